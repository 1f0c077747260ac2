"""MXFP8 (OCP microscaling: E4M3 values, one power-of-two UE8M0 scale per 32 elements) quantisation, GEMM and
a linear layer built from them.

A tensor is quantised in up to two directions because a block-scaled MMA needs the scales along the reduced
dimension of each GEMM:

==========  ===========================  ==============================
GEMM        A operand                    B operand
==========  ===========================  ==============================
fprop       x   row-wise  (over in)      W   row-wise  (over in)
dgrad       dy  row-wise  (over out)     W   col-wise  (over out)
wgrad       dy  col-wise  (over tokens)  x   col-wise  (over tokens)
==========  ===========================  ==============================

so the forward pass stores the *col-wise fp8* copy of ``x`` for the backward pass instead of the bf16
activation, and a weight is quantised (both directions) once per optimizer step.

``quantize_mxfp8_ref`` / ``dequantize_mxfp8_ref`` restate the rounding rules in plain PyTorch (the numerics
oracle and the CPU path).  Counterpart of the reference's fp8 recipes
(primus/backends/megatron/core/extensions/primus_turbo.py float8 linear; MXFP8 recipe
primus/backends/megatron/patches/args/rocm_arg_validation.py).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

BLOCK = 32
TILE = 128


@dataclass
class MXFP8Tensor:
    shape: tuple
    q_row: Optional[torch.Tensor] = None   # uint8 view of E4M3 [R, C], scales along C
    sf_row: Optional[torch.Tensor] = None  # uint8 [R * C / 32] (512-byte block layout, MN = R)
    q_col: Optional[torch.Tensor] = None   # uint8 [R, C], scales along R
    sf_col: Optional[torch.Tensor] = None  # uint8 [R * C / 32] (block layout, MN = C)


def sf_offsets(mn: torch.Tensor, kblk: torch.Tensor, k_groups: int) -> torch.Tensor:
    """Byte offset of the scale of row ``mn`` and 32-element block ``kblk`` in the 512-byte block layout."""
    return ((mn // 128) * k_groups + kblk // 4) * 512 + (mn % 32) * 16 + ((mn % 128) // 32) * 4 + kblk % 4


def _e8m0(amax: torch.Tensor) -> torch.Tensor:
    v = (amax.float() * torch.tensor(1.0 / 448.0, dtype=torch.float32, device=amax.device))
    bits = v.view(torch.int32)
    e = (bits >> 23) & 0xFF
    e = e + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    e = e.clamp(0, 254)
    return torch.where(amax == 0, torch.zeros_like(e), e)


# Scaling recipe of ``quantize_mxfp8`` (set by ``ops.gemm.set_fp8_recipe``).  All recipes store E4M3 values with UE8M0
# exponents in the MXFP8 layout, so every GEMM runs on the same block-scaled kernel; they differ in which elements share
# an exponent and where it comes from:
#   "mxfp8"       every 32 elements along the reduced dimension, from their own maximum
#   "tensorwise"  the whole tensor, from its current maximum ("current scaling")
#   "delayed"     the whole tensor, from the maxima recorded in earlier steps (``DelayedScaling``)
#   "blockwise"   activations / gradients: every 1 x 128 vector along the reduced dimension; weights: 128 x 128 tiles
#   "mxfp4"       MXFP4 numerics (E2M1 values, one UE8M0 scale per 32 elements) in FP8 storage: values are rounded to
#                 the E2M1 grid and kept as the E4M3 bytes of the same numbers, so convergence under 4-bit operands can
#                 be studied on the FP8 tensor-core path (FP8 throughput, not the 2x of packed 4-bit operands)
SCALING = "mxfp8"
TENSORWISE = False      # kept in step with SCALING == "tensorwise" for callers that read the old switch


class DelayedScaling:
    """State of the delayed-scaling recipe: for every (tensor role) slot the maximum seen since the last roll
    (``amax_now``, written by the quantiser with an atomic maximum), a history of the last ``history_len`` rolled
    maxima, and the maximum the next quantisations scale by (``scale_amax``: the largest or the most recent history
    entry, times ``2^margin``).  ``roll()`` runs once per optimizer step, entirely on the device; with a process
    group the rolled maxima are first max-reduced over it, so ranks holding shards of one tensor use one scale.

    Behaviour of Transformer-Engine's ``DelayedScaling(margin, amax_history_len, amax_compute_algo)`` as driven by the
    reference's ``--fp8-amax-history-len / --fp8-amax-compute-algo / --fp8-margin`` arguments (the ``delayed`` entry of
    ``fp8_recipe`` in primus/configs/modules/megatron/trainer_base.yaml), with power-of-two scales."""

    def __init__(self, history_len: int = 1, algo: str = "most_recent", margin: int = 0, capacity: int = 1024):
        assert algo in ("max", "most_recent"), algo
        self.history_len, self.algo, self.margin = max(1, int(history_len)), algo, int(margin)
        self.capacity = capacity
        self.slots: dict = {}
        self.amax_now = self.history = self.scale_amax = None

    def _allocate(self, device):
        self.amax_now = torch.zeros(self.capacity, dtype=torch.float32, device=device)
        self.scale_amax = torch.zeros(self.capacity, dtype=torch.float32, device=device)
        self.history = torch.zeros(self.history_len, self.capacity, dtype=torch.float32, device=device)

    def slot(self, key, device) -> int:
        i = self.slots.get(key)
        if i is None:
            i = self.slots[key] = len(self.slots)
            if self.amax_now is None:
                self._allocate(device)
            elif i >= self.capacity:
                old = (self.amax_now, self.scale_amax, self.history)
                self.capacity *= 2
                self._allocate(device)
                n = old[0].numel()
                self.amax_now[:n], self.scale_amax[:n], self.history[:, :n] = old
        return i

    def roll(self, group=None) -> None:
        """Push the maxima of the step that just ended into the history and derive the next step's scales."""
        if self.amax_now is None:
            return
        if group is not None and torch.distributed.get_world_size(group) > 1:
            torch.distributed.all_reduce(self.amax_now, op=torch.distributed.ReduceOp.MAX, group=group)
        seen = self.amax_now > 0            # a slot not used this step keeps its history
        rolled = torch.roll(self.history, 1, 0)
        rolled[0] = self.amax_now
        self.history.copy_(torch.where(seen[None, :], rolled, self.history))
        pick = self.history.amax(0) if self.algo == "max" else self.history[0]
        self.scale_amax.copy_(pick * float(2.0 ** self.margin))
        self.amax_now.zero_()

    def state_dict(self) -> dict:
        if self.amax_now is None:
            return {}
        return {"keys": list(self.slots), "history": self.history[:, :len(self.slots)].cpu(),
                "scale_amax": self.scale_amax[:len(self.slots)].cpu()}


DELAYED: Optional[DelayedScaling] = None


def _e8m0_fp4(amax: torch.Tensor) -> torch.Tensor:
    """Exponent that brings a block maximum to at most 6, the largest E2M1 magnitude."""
    v = (amax.float() * torch.tensor(1.0 / 6.0, dtype=torch.float32, device=amax.device))
    bits = v.view(torch.int32)
    e = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return torch.where(amax == 0, torch.zeros_like(e), e.clamp(0, 254))


_E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def round_to_e2m1(v: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even onto the E2M1 grid (saturating at +-6)."""
    a = v.abs()
    idx = torch.zeros_like(a, dtype=torch.int64)
    for j in range(7):
        mid = 0.5 * (_E2M1_GRID[j] + _E2M1_GRID[j + 1])
        idx += (a > mid) if j % 2 == 0 else (a >= mid)      # a tie goes to the code with an even mantissa bit
    grid = torch.tensor(_E2M1_GRID, dtype=torch.float32, device=v.device)
    return torch.copysign(grid[idx], v)


def _block_exponents(xf: torch.Tensor, direction: str, scaling: str, is_weight: bool, e_all) -> torch.Tensor:
    """UE8M0 exponent of every 32-block of ``xf`` [R, C]: [R, C/32] ("row") or [R/32, C] ("col")."""
    R, C = xf.shape
    a = xf.abs()
    if direction == "row":
        shape = (R, C // BLOCK)
        if scaling in ("tensorwise", "delayed"):
            return e_all.expand(shape).contiguous()
        if scaling == "blockwise" and is_weight:
            t = a.view(R // TILE, TILE, C // TILE, TILE).amax((1, 3))                       # [R/128, C/128]
            return _e8m0(t).repeat_interleave(TILE, 0).repeat_interleave(TILE // BLOCK, 1)
        if scaling == "blockwise":
            return _e8m0(a.view(R, C // TILE, TILE).amax(-1)).repeat_interleave(TILE // BLOCK, 1)
        if scaling == "mxfp4":
            return _e8m0_fp4(a.view(R, C // BLOCK, BLOCK).amax(-1))
        return _e8m0(a.view(R, C // BLOCK, BLOCK).amax(-1))
    shape = (R // BLOCK, C)
    if scaling in ("tensorwise", "delayed"):
        return e_all.expand(shape).contiguous()
    if scaling == "blockwise" and is_weight:
        t = a.view(R // TILE, TILE, C // TILE, TILE).amax((1, 3))
        return _e8m0(t).repeat_interleave(TILE // BLOCK, 0).repeat_interleave(TILE, 1)
    if scaling == "blockwise":
        return _e8m0(a.view(R // TILE, TILE, C).amax(1)).repeat_interleave(TILE // BLOCK, 0)
    if scaling == "mxfp4":
        return _e8m0_fp4(a.view(R // BLOCK, BLOCK, C).amax(1))
    return _e8m0(a.view(R // BLOCK, BLOCK, C).amax(1))


def quantize_mxfp8_ref(x: torch.Tensor, rowwise: bool = True, colwise: bool = True,
                       tensorwise: Optional[bool] = None, scaling: Optional[str] = None, is_weight: bool = False,
                       scale_amax: Optional[torch.Tensor] = None) -> MXFP8Tensor:
    """Plain-PyTorch statement of every recipe's rounding rules.  ``scale_amax`` (delayed scaling): the maximum the
    scale is derived from; zero or None falls back to the tensor's own maximum."""
    R, C = x.shape
    assert R % TILE == 0 and C % TILE == 0
    xf = x.float()
    scaling = ("tensorwise" if tensorwise else "mxfp8") if tensorwise is not None and scaling is None else (scaling or SCALING)
    e_all = None
    if scaling in ("tensorwise", "delayed"):
        amax = xf.abs().amax().reshape(1)
        if scaling == "delayed" and scale_amax is not None:
            sa = scale_amax.reshape(1).to(amax)
            amax = torch.where(sa > 0, sa, amax)
        e_all = _e8m0(amax)
    out = MXFP8Tensor(shape=(R, C))
    dev = x.device
    for direction in ("row", "col"):
        if (direction == "row" and not rowwise) or (direction == "col" and not colwise):
            continue
        e = _block_exponents(xf, direction, scaling, is_weight, e_all)
        inv = ((254 - e).clamp(min=1) << 23).view(torch.float32)
        if direction == "row":
            q = (xf.view(R, C // BLOCK, BLOCK) * inv[..., None]).reshape(R, C)
            mn = torch.arange(R, device=dev)[:, None].expand(R, C // BLOCK)
            kb = torch.arange(C // BLOCK, device=dev)[None, :].expand(R, C // BLOCK)
            off = sf_offsets(mn, kb, C // TILE)
        else:
            q = (xf.view(R // BLOCK, BLOCK, C) * inv[:, None, :]).reshape(R, C)
            mn = torch.arange(C, device=dev)[None, :].expand(R // BLOCK, C)
            kb = torch.arange(R // BLOCK, device=dev)[:, None].expand(R // BLOCK, C)
            off = sf_offsets(mn, kb, R // TILE)
        if scaling == "mxfp4":
            q = round_to_e2m1(q)
        q8 = q.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
        sf = torch.zeros(R * C // BLOCK, dtype=torch.uint8, device=dev)
        sf[off.reshape(-1)] = e.reshape(-1).to(torch.uint8)
        if direction == "row":
            out.q_row, out.sf_row = q8, sf
        else:
            out.q_col, out.sf_col = q8, sf
    return out


def dequantize_mxfp8_ref(q: torch.Tensor, sf: torch.Tensor, colwise: bool) -> torch.Tensor:
    R, C = q.shape
    dev = q.device
    r = torch.arange(R, device=dev)[:, None].expand(R, C)
    c = torch.arange(C, device=dev)[None, :].expand(R, C)
    off = sf_offsets(c, r // BLOCK, R // TILE) if colwise else sf_offsets(r, c // BLOCK, C // TILE)
    e = sf[off.reshape(-1)].view(R, C).float()
    return q.view(torch.float8_e4m3fn).float() * torch.exp2(e - 127.0)


def quantize_mxfp8(x: torch.Tensor, rowwise: bool = True, colwise: bool = True, tensorwise: Optional[bool] = None,
                   scaling: Optional[str] = None, is_weight: bool = False, slot_key=None) -> MXFP8Tensor:
    """bf16 [R, C] (R, C multiples of 128) -> FP8 values + block exponents in the requested directions.

    ``scaling`` (default: the module recipe ``SCALING``) picks the recipe; ``tensorwise=True/False`` is shorthand for
    "tensorwise" / "mxfp8".  ``is_weight`` matters to "blockwise" (128 x 128 tiles instead of 1 x 128 vectors);
    ``slot_key`` names the tensor's role for "delayed" (a tensor without a key is scaled by its current maximum)."""
    if scaling is None:
        scaling = SCALING if tensorwise is None else ("tensorwise" if tensorwise else "mxfp8")
    delayed_slot = None
    if scaling == "delayed":
        if DELAYED is None or slot_key is None:
            scaling = "tensorwise"
        else:
            delayed_slot = DELAYED.slot(slot_key, x.device)
    if not x.is_cuda:
        if delayed_slot is not None:
            out = quantize_mxfp8_ref(x, rowwise, colwise, None, "delayed", is_weight,
                                     DELAYED.scale_amax[delayed_slot])
            DELAYED.amax_now[delayed_slot] = torch.maximum(DELAYED.amax_now[delayed_slot], x.float().abs().amax())
            return out
        return quantize_mxfp8_ref(x, rowwise, colwise, None, scaling, is_weight)
    R, C = x.shape
    assert R % TILE == 0 and C % TILE == 0, "FP8 quantisation needs dimensions that are multiples of 128"
    x = x.contiguous()
    if x.dtype != torch.bfloat16:
        x = x.bfloat16()
    dev = x.device
    out = MXFP8Tensor(shape=(R, C))
    if rowwise:
        out.q_row = torch.empty(R, C, dtype=torch.uint8, device=dev)
        out.sf_row = torch.empty(R * C // BLOCK, dtype=torch.uint8, device=dev)
    if colwise:
        out.q_col = torch.empty(R, C, dtype=torch.uint8, device=dev)
        out.sf_col = torch.empty(R * C // BLOCK, dtype=torch.uint8, device=dev)
    if delayed_slot is not None:
        _lib.call("quant_fp8_delayed", x, R, C, DELAYED.amax_now[delayed_slot:], DELAYED.scale_amax[delayed_slot:],
                  out.q_row, out.sf_row, out.q_col, out.sf_col)
    elif scaling == "tensorwise":
        amax = torch.empty(1, dtype=torch.float32, device=dev)
        _lib.call("quant_fp8_tensorwise", x, R, C, amax, out.q_row, out.sf_row, out.q_col, out.sf_col)
    elif scaling == "blockwise":
        _lib.call("quant_fp8_blockwise", x, R, C, int(is_weight), out.q_row, out.sf_row, out.q_col, out.sf_col)
    elif scaling == "mxfp4":
        _lib.call("quant_mxfp4_as_fp8", x, R, C, out.q_row, out.sf_row, out.q_col, out.sf_col)
    else:
        _lib.call("quant_mxfp8", x, R, C, out.q_row, out.sf_row, out.q_col, out.sf_col)
    return out


def swiglu_quantize_mxfp8(h1: torch.Tensor, clamp: float = 0.0, rowwise: bool = True, colwise: bool = False) -> MXFP8Tensor:
    """MXFP8 of ``silu(gate) * up`` for ``h1 = [gate | up]`` [T, 2I] without materialising the bf16 activation
    (values identical to quantising the un-fused SwiGLU output)."""
    T, I2 = h1.shape
    I = I2 // 2
    dev = h1.device
    out = MXFP8Tensor(shape=(T, I))
    if rowwise:
        out.q_row = torch.empty(T, I, dtype=torch.uint8, device=dev)
        out.sf_row = torch.empty(T * I // BLOCK, dtype=torch.uint8, device=dev)
    if colwise:
        out.q_col = torch.empty(T, I, dtype=torch.uint8, device=dev)
        out.sf_col = torch.empty(T * I // BLOCK, dtype=torch.uint8, device=dev)
    _lib.call("swiglu_quant_mxfp8", h1, T, I, float(clamp), out.q_row, out.sf_row, out.q_col, out.sf_col)
    return out


def swiglu_bwd_quantize_mxfp8(h1: torch.Tensor, dact: torch.Tensor, clamp: float = 0.0) -> MXFP8Tensor:
    """MXFP8 (both directions) of the SwiGLU input gradient ``[dgate | dup]`` [T, 2I] from ``h1`` and ``dact`` [T, I]."""
    T, I2 = h1.shape
    I = I2 // 2
    dev = h1.device
    out = MXFP8Tensor(shape=(T, I2))
    out.q_row = torch.empty(T, I2, dtype=torch.uint8, device=dev)
    out.sf_row = torch.empty(T * I2 // BLOCK, dtype=torch.uint8, device=dev)
    out.q_col = torch.empty(T, I2, dtype=torch.uint8, device=dev)
    out.sf_col = torch.empty(T * I2 // BLOCK, dtype=torch.uint8, device=dev)
    _lib.call("swiglu_bwd_quant_mxfp8", h1, dact, T, I, float(clamp), out.q_row, out.sf_row, out.q_col, out.sf_col)
    return out


def dequantize_mxfp8(q: torch.Tensor, sf: torch.Tensor, colwise: bool) -> torch.Tensor:
    if not q.is_cuda:
        return dequantize_mxfp8_ref(q, sf, colwise)
    R, C = q.shape
    out = torch.empty(R, C, dtype=torch.float32, device=q.device)
    _lib.call("dequant_mxfp8", q, sf, R, C, int(colwise), out)
    return out


# CTA-pair kernel (256 x 256 tiles, csrc/gemm_mxfp8_2cta.cu) for problems with at least this many rows / columns: each
# CTA of a pair reads half of B, which takes the shared-memory operand reads off the critical path of the one-CTA kernel
# (+2 % on single GEMMs in bursts, +0.5 % on the power-capped Llama-3.1-8B step, same numerics).  PRIMUS_B200_TWO_CTA_MIN_DIM overrides the
# threshold; 0 disables the kernel.
_env_min = os.environ.get("PRIMUS_B200_TWO_CTA_MIN_DIM")
TWO_CTA_MIN_DIM: Optional[int] = (int(_env_min) or None) if _env_min else 256


def launch_gemm(a_q, a_sf, b_q, b_sf, out, M: int, N: int, K: int, a_mn: bool, b_mn: bool, mode: int,
                block_n: Optional[int] = None, max_ctas: int = 0, two_cta: Optional[bool] = None) -> None:
    dev = out.device
    if two_cta is None:
        two_cta = TWO_CTA_MIN_DIM is not None and M >= TWO_CTA_MIN_DIM and N >= TWO_CTA_MIN_DIM and block_n in (None, 256)
    if two_cta:
        _lib.call("gemm_mxfp8_2cta", a_q, a_sf, b_q, b_sf, out, M, N, K, a_q.stride(0), b_q.stride(0), out.stride(0),
                  int(a_mn), int(b_mn), mode, max_ctas, _lib.status_word(dev))
        return
    if block_n is None:
        block_n = 256 if N >= 256 else 128
    _lib.call("gemm_mxfp8", a_q, a_sf, b_q, b_sf, out, M, N, K, a_q.stride(0), b_q.stride(0), out.stride(0),
              int(a_mn), int(b_mn), mode, block_n, max_ctas, _lib.status_word(dev))


def gemm_mxfp8(a_q, a_sf, b_q, b_sf, M: int, N: int, K: int, a_mn: bool = False, b_mn: bool = False,
               out: Optional[torch.Tensor] = None, accumulate: bool = False, out_dtype=torch.bfloat16,
               block_n: Optional[int] = None, two_cta: Optional[bool] = None) -> torch.Tensor:
    """D[M, N] (=|+=) A . B^T with MXFP8 operands.  ``a_q``: [M, K] (``a_mn`` False) or [K, M] (True); likewise
    ``b_q`` with N.  fp32 ``out`` with ``accumulate`` adds into it (main-grad accumulation)."""
    dev = a_q.device
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=dev)
    mode = 0 if out.dtype == torch.bfloat16 else (2 if accumulate else 1)
    launch_gemm(a_q, a_sf, b_q, b_sf, out, M, N, K, a_mn, b_mn, mode, block_n, 0, two_cta)
    return out


# ----------------------------------------------------------------------------------------------
class _WeightCache:
    """Quantised copies of a weight, refreshed when the parameter has been updated (version counter)."""

    def __init__(self):
        self.store: dict = {}

    def get(self, w: torch.Tensor) -> MXFP8Tensor:
        key = id(w)
        ver = w._version
        hit = self.store.get(key)
        if hit is not None and hit[0] == ver and hit[1] == w.data_ptr():
            return hit[2]
        q = quantize_mxfp8(w.detach(), True, True)
        self.store[key] = (ver, w.data_ptr(), q)
        return q

    def clear(self):
        self.store.clear()


WEIGHT_CACHE = _WeightCache()


class LinearMXFP8Fn(torch.autograd.Function):
    """y = x W^T with all three GEMMs in MXFP8 (fp32 accumulation; wgrad accumulates into ``w.main_grad`` when the
    parameter has one)."""

    @staticmethod
    def forward(ctx, x, w):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        T, K = x2.shape
        N = w.shape[0]
        xq = quantize_mxfp8(x2, True, w.requires_grad)
        wq = WEIGHT_CACHE.get(w)
        y = gemm_mxfp8(xq.q_row, xq.sf_row, wq.q_row, wq.sf_row, T, N, K)
        ctx.save_for_backward(xq.q_col if xq.q_col is not None else torch.empty(0),
                              xq.sf_col if xq.sf_col is not None else torch.empty(0))
        ctx.w_ref = w
        ctx.dims = (T, N, K, shape)
        return y.view(*shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x_col, x_sf = ctx.saved_tensors
        w = ctx.w_ref
        T, N, K, shape = ctx.dims
        dy2 = dy.reshape(T, N)
        need_w = ctx.needs_input_grad[1]
        dyq = quantize_mxfp8(dy2, ctx.needs_input_grad[0], need_w)
        dx = None
        if ctx.needs_input_grad[0]:
            wq = WEIGHT_CACHE.get(w)
            # dx[T, K] = dy[T, N] . W[N, K]: B is W stored [K_red = N, N_out = K]
            dx = gemm_mxfp8(dyq.q_row, dyq.sf_row, wq.q_col, wq.sf_col, T, K, N, b_mn=True).view(shape)
        dw = None
        if need_w:
            mg = getattr(w, "main_grad", None)
            tgt = mg if mg is not None else torch.empty(N, K, dtype=torch.float32, device=dy.device)
            # dW[N, K] = dy^T . x: A is dy stored [K_red = T, M = N], B is x stored [K_red = T, N_out = K]
            gemm_mxfp8(dyq.q_col, dyq.sf_col, x_col, x_sf, N, K, T, a_mn=True, b_mn=True, out=tgt,
                       accumulate=mg is not None)
            if mg is None:
                dw = tgt.to(w.dtype)
            else:
                cb = getattr(w, "_grad_ready_cb", None)
                if cb is not None:
                    cb(w)
        return dx, dw


def linear_mxfp8(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """MXFP8 linear; falls back to the reference arithmetic (dequantised operands) on CPU tensors."""
    if not x.is_cuda:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        xq = quantize_mxfp8_ref(x2, True, False)
        wq = quantize_mxfp8_ref(w.detach(), True, False)
        y = dequantize_mxfp8_ref(xq.q_row, xq.sf_row, False) @ dequantize_mxfp8_ref(wq.q_row, wq.sf_row, False).t()
        return y.to(x.dtype).view(*shape[:-1], w.shape[0])
    return LinearMXFP8Fn.apply(x, w)
