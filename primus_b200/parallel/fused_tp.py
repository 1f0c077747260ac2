"""Tensor-parallel GEMMs fused with their collective (``csrc/gemm_tp_fused.cu``).

``ag_gemm(x_shard, w)``  : ``all_gather(x_shard) @ w.T``   -> (out [T, N], gathered [T, K])
``gemm_rs(x, w)``        : ``reduce_scatter(x @ w.T)``     -> out [T/tp, N]

Both run as ONE persistent kernel in which communication CTAs move peer data over NVLink with P2P
loads while GEMM CTAs (tcgen05) work on the tiles whose operands / destinations are ready.  The
NCCL pair (``all_gather_into_tensor`` + GEMM, GEMM + ``reduce_scatter_tensor``) stays available as the
baseline (``fused=False``) and is what CPU/gloo runs use.

Workspaces (symmetric activation shard, symmetric partial-product buffer, local gather buffer, fp32
accumulator, counters) are cached per (group, shape): the tensors returned by ``ag_gemm`` (``gathered``)
are views of such a workspace and are valid until the next fused call with the same shape.

Which GEMMs use which form follows the reference's user-buffer table
(primus/backends/transformer_engine/pytorch/module/base.py:141-159): all-gather overlap for
qkv/fc1 fprop and proj/fc2 dgrad, reduce-scatter overlap for proj/fc2 fprop and qkv/fc1 dgrad.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib, gemm as gemm_ops
from . import tensor_parallel as tpc
from .symm_mem import SymmetricBuffer

COMM_CTAS = int(os.environ.get("PRIMUS_B200_TP_COMM_CTAS", "16"))
# Fused kernels on/off (config key ``tp_comm_overlap``); off = NCCL collective + GEMM.
# all-gather -> GEMM fused kernel (column-parallel layers and the data gradients of row-parallel ones)
ENABLED = os.environ.get("PRIMUS_B200_TP_FUSED", "0") == "1"
# GEMM -> reduce-scatter fused kernel (row-parallel layers); measured slower than GEMM + NCCL at tp = 8, so it has a
# switch of its own
ENABLED_RS = os.environ.get("PRIMUS_B200_TP_FUSED_RS", "0") == "1"


class _Instance:
    """Everything one (mode, M, N, K) fused op needs; flag slots and epochs are private to it."""
    _next_slot = 0

    def __init__(self, ctx: "FusedTPContext", mode: int, M: int, N: int, K: int):
        self.mode, self.M, self.N, self.K = mode, M, N, K
        tp = ctx.tp
        dev = ctx.device
        self.epoch = 0
        self.slot = _Instance._next_slot
        _Instance._next_slot += 1
        assert self.slot < 60, "too many distinct fused TP shapes"
        # chunk progress + reads done + published prefixes (3 x 8), accumulator row-block counts (256), tiles done per
        # row block of every chunk (8 x 256); monotonic over epochs, zeroed once
        self.counters = torch.zeros(3 * 8 + 256 + 8 * 256, dtype=torch.int32, device=dev)
        Tl = M // tp
        if mode == 0:
            self.sym = SymmetricBuffer(Tl * K * 2, ctx.group, dev)       # activation shard of every rank
            self.gather = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
            self.acc = None
            self.out_rs = None
        else:
            self.sym = SymmetricBuffer(M * N * 2, ctx.group, dev)        # partial product of every rank
            self.gather = None
            self.acc = torch.empty(Tl, N, dtype=torch.bfloat16, device=dev)   # sum of the remote partials of my rows
        # flag slot range of this instance inside the symmetric buffer's own flag area
        self.peer_payload = (ctypes.c_long * 8)(*[self.sym.peer_ptr(r) for r in range(tp)], *([0] * (8 - tp)))
        self.peer_flags = (ctypes.c_long * 8)(*[self.sym.peer_ptr(r) + self.sym.nbytes for r in range(tp)],
                                               *([0] * (8 - tp)))
        self.local_flags = self.sym.flags


class FusedTPContext:
    def __init__(self, group):
        self.group = group
        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._inst: dict = {}

    def instance(self, mode: int, M: int, N: int, K: int) -> _Instance:
        key = (mode, M, N, K)
        inst = self._inst.get(key)
        if inst is None:
            inst = _Instance(self, mode, M, N, K)
            self._inst[key] = inst
        return inst

    def supported(self, M: int, N: int, K: int) -> bool:
        return self.tp >= 2 and M % self.tp == 0 and (M // self.tp) % 128 == 0 and K % 8 == 0 and N % 8 == 0


_CTX: dict = {}


def get_context(group) -> FusedTPContext:
    key = id(group)
    if key not in _CTX:
        _CTX[key] = FusedTPContext(group)
    return _CTX[key]


def _comm_ctas(ctx, inst) -> int:
    """Copy CTAs of a launch: the count (a multiple of 8, at most 48) that balances the two halves of the kernel under a
    simple model -- a copy CTA moves ~17.5 GB/s (one thread drives its ring of bulk copies), all of them together at
    most ~700 GB/s over NVLink, and the GEMM runs at ~1.4 PFLOP/s on the SMs that are left.  ``PRIMUS_B200_TP_COMM_CTAS``
    fixes the count; TP = 2 keeps the default, which was measured."""
    if "PRIMUS_B200_TP_COMM_CTAS" in os.environ or ctx.tp == 2:
        return COMM_CTAS
    width = inst.K if inst.mode == 0 else inst.N      # gathered activations [M, K] / partial products [M, N]
    nbytes = (ctx.tp - 1) / ctx.tp * inst.M * width * 2
    flops = 2.0 * inst.M * inst.N * inst.K
    best, best_t = COMM_CTAS, float("inf")
    # the reduce-scatter's copy CTAs also add the copies (all threads, two barriers per piece): fewer bytes per CTA and
    # never fewer than 16 of them (8 measured 0.67x of GEMM + NCCL on the TP = 4 FC2 shape)
    rate = 17.5e9 if inst.mode == 0 else 12e9
    for c in ((8, 16, 24, 32, 40, 48) if inst.mode == 0 else (16, 24, 32, 40, 48)):
        t = max(nbytes / min(c * rate, 700e9), flops / (1.4e15 * (148 - c) / 148))
        if t < best_t * 0.97:     # prefer fewer copy CTAs unless more of them buy at least 3 %
            best, best_t = c, t
    return best


def _launch(ctx, inst, A, B, D, b_mn, out_rs=None):
    null = ctypes.c_void_p(0)
    inst.epoch += 1
    lib = _lib.require()
    fn = lib.pb_gemm_tp_fused
    fn.restype = ctypes.c_int
    vp = ctypes.c_void_p
    _lib.LAUNCH_COUNT += 1
    rc = fn(ctypes.c_int(inst.mode), ctypes.c_int(ctx.tp), ctypes.c_int(ctx.rank), ctypes.c_int(inst.epoch),
            ctypes.c_int(_comm_ctas(ctx, inst)), vp(A.data_ptr()), vp(B.data_ptr()), vp(D.data_ptr()), ctypes.c_int(inst.M),
            ctypes.c_int(inst.N), ctypes.c_int(inst.K), ctypes.c_long(B.stride(0)), ctypes.c_int(int(b_mn)),
            inst.peer_payload if inst.mode == 0 else null,
            vp(inst.gather.data_ptr()) if inst.mode == 0 else null,
            inst.peer_payload if inst.mode == 1 else null,
            vp(inst.acc.data_ptr()) if inst.mode == 1 else null,
            vp(out_rs.data_ptr()) if out_rs is not None else null,
            vp(inst.counters.data_ptr()), inst.peer_flags, vp(inst.local_flags.data_ptr()),
            vp(_lib.status_word(ctx.device).data_ptr()), _lib.stream_ptr())
    if rc != 0:
        raise _lib.NativeLibraryError(f"pb_gemm_tp_fused failed with code {rc}")


# Under the MXFP8 recipe the all-gather of a sequence-parallel activation moves its quantised copy (E4M3 values + UE8M0
# block scales: 0.52 x the bytes of bf16 per direction) and every rank quantises only its own shard; blocks never
# straddle shards because a shard is a multiple of 128 rows, so the gathered copy is bit-identical to quantising the
# gathered tensor.
QUANTIZED_GATHER = True

_FALLBACK_LOGGED: set = set()


def _quantized_gather_ok(x_shard, w, b_mn: bool) -> bool:
    if not (QUANTIZED_GATHER and x_shard.is_cuda and gemm_ops.fp8_recipe() == "mxfp8"):
        return False
    if gemm_ops.WGRAD_STORE.current is not None:      # deferred weight-gradient GEMMs would outlive the placeholder table
        return False
    if x_shard.dtype != torch.bfloat16 or not x_shard.is_contiguous() or not w.is_contiguous():
        return False
    if getattr(w, "_fp8_exempt", False) or getattr(x_shard, "_fp8_exempt", False):
        return False
    Tl, K = x_shard.shape
    N = w.shape[1] if b_mn else w.shape[0]
    return Tl % 128 == 0 and K % 128 == 0 and N % 128 == 0


def all_gather_quantized(x_shard: torch.Tensor, group, row: bool = True, col: bool = False) -> torch.Tensor:
    """All-gather (dim 0) of the MXFP8 copies of ``x_shard`` [Tl, K].  Returns a bf16 placeholder [T, K] whose contents
    are never written: its quantised copies are registered with ``ops.gemm``, so FP8-eligible GEMMs that take it as an
    operand use them.  ``row``: blocks along K (forward / data-gradient operand); ``col``: blocks along the tokens
    (weight-gradient operand)."""
    from ..ops import fp8

    tp = dist.get_world_size(group)
    Tl, K = x_shard.shape
    T = Tl * tp
    q = fp8.quantize_mxfp8(x_shard, row, col, scaling="mxfp8")
    full = fp8.MXFP8Tensor(shape=(T, K))
    if row:
        full.q_row = tpc.all_gather_dim0(q.q_row, group)
        full.sf_row = tpc.all_gather_dim0(q.sf_row, group)           # [Tl/128][K/128][512]: row blocks are outermost
    if col:
        full.q_col = tpc.all_gather_dim0(q.q_col, group)
        # column-direction scales are laid out [K/128][Tl/128][512]: the shards interleave in the middle dimension
        sf = tpc.all_gather_dim0(q.sf_col.view(1, K // 128, Tl // 128, 512), group)
        full.sf_col = sf.permute(1, 0, 2, 3).contiguous().view(-1)
    placeholder = torch.empty(T, K, dtype=torch.bfloat16, device=x_shard.device)
    gemm_ops.register_quantized(placeholder, full, pinned=True)
    return placeholder


def _note_fallback(kind: str, reason: str) -> None:
    """One log line per (kernel, reason) when a fused kernel was requested and the NCCL composition runs instead."""
    if (kind, reason) not in _FALLBACK_LOGGED:
        _FALLBACK_LOGGED.add((kind, reason))
        import logging

        logging.getLogger("primus_b200").warning("fused %s requested but not used: %s; running NCCL + GEMM", kind, reason)
        if not dist.is_initialized() or dist.get_rank() == 0:
            print(f"[fused-tp] {kind} requested but not used: {reason}; running NCCL + GEMM", flush=True)


def ag_gemm(x_shard: torch.Tensor, w: torch.Tensor, group, b_mn: bool = False, fused: bool = True,
            gather_col: bool = False):
    """Returns (all_gather(x_shard) @ W^T, gathered x). ``w``: [N, K] or, with ``b_mn``, [K, N].  Under the MXFP8
    recipe the gathered tensor may be a placeholder that only carries quantised copies (``all_gather_quantized``);
    ``gather_col`` asks for the token-direction copy as well (the caller feeds it to a weight-gradient GEMM)."""
    tp = dist.get_world_size(group)
    if _quantized_gather_ok(x_shard, w, b_mn):
        g = all_gather_quantized(x_shard, group, row=True, col=gather_col)
        return gemm_ops.gemm(g, w, b_mn=b_mn), g
    Tl, K = x_shard.shape
    M = Tl * tp
    N = w.shape[1] if b_mn else w.shape[0]
    # the fused kernels are bf16: under an FP8 recipe the collective stays on NCCL and the GEMM runs in FP8
    if fused and gemm_ops.fp8_recipe() is not None:
        _note_fallback("all-gather -> GEMM", f"the fused kernel is bf16 and fp8_recipe is {gemm_ops.fp8_recipe()!r}")
        fused = False
    ctx = get_context(group) if (fused and x_shard.is_cuda) else None
    if fused and x_shard.is_cuda and (ctx is None or not ctx.supported(M, N, K)):
        _note_fallback("all-gather -> GEMM", "no peer-memory context for this group" if ctx is None else
                       f"shape M={M} N={N} K={K} is not supported")
    if ctx is None or not ctx.supported(M, N, K):
        g = tpc.all_gather_dim0(x_shard, group)
        return gemm_ops.gemm(g, w, b_mn=b_mn), g
    inst = ctx.instance(0, M, N, K)
    inst.sym.local(torch.bfloat16, Tl * K).view(Tl, K).copy_(x_shard)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x_shard.device)
    _launch(ctx, inst, inst.gather, w, out, b_mn)
    return out, inst.gather


def gemm_rs(x: torch.Tensor, w: torch.Tensor, group, b_mn: bool = False, fused: bool = True) -> torch.Tensor:
    """Returns reduce_scatter(x @ W^T) over dim 0."""
    tp = dist.get_world_size(group)
    M, K = x.shape
    N = w.shape[1] if b_mn else w.shape[0]
    if fused and gemm_ops.fp8_recipe() is not None:
        _note_fallback("GEMM -> reduce-scatter", f"the fused kernel is bf16 and fp8_recipe is {gemm_ops.fp8_recipe()!r}")
        fused = False
    ctx = get_context(group) if (fused and x.is_cuda) else None
    # N % 128: accumulator pieces are whole fractions of a 128-row block; at most 256 row blocks per rank
    if fused and x.is_cuda and (ctx is None or not ctx.supported(M, N, K) or N % 128 or M // tp > 32768
                                or not x.is_contiguous()):
        _note_fallback("GEMM -> reduce-scatter", "no peer-memory context for this group" if ctx is None else
                       f"shape M={M} N={N} K={K} is not supported")
    if ctx is None or not ctx.supported(M, N, K) or N % 128 or M // tp > 32768 or not x.is_contiguous():
        return tpc.reduce_scatter_dim0(gemm_ops.gemm(x, w, b_mn=b_mn), group)
    inst = ctx.instance(1, M, N, K)
    partial = inst.sym.local(torch.bfloat16, M * N).view(M, N)
    out = torch.empty(M // tp, N, dtype=torch.bfloat16, device=x.device)
    _launch(ctx, inst, x, w, partial, b_mn, out_rs=out)
    return out
