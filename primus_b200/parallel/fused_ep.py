"""Expert parallelism with the dispatch / combine all-to-all fused into the expert GEMMs
(``csrc/moe_fused.cu``) over symmetric memory.

Per MoE layer and direction the sequence is::

    plan_count -> barrier -> plan_assign, publish tokens -> barrier -> [dispatch + GEMM1] -> SwiGLU x prob
               -> [GEMM2 + combine pull] -> local top-k sum

* no host synchronisation: counts, the padded expert-major layout of every rank and the row of every
  token copy are computed on the device from a count table exchanged with P2P stores;
* buffers are sized for ``capacity_factor x T x k`` routed rows per rank (default: the worst case,
  ``ep x T x k``); an overflow raises the device status ``PB_ERR_CAPACITY`` instead of corrupting memory;
* the backward pass reuses the same two kernels with the roles swapped: the gradient of the combined
  output is *dispatched* (gather + data-gradient GEMM of FC2), the data gradient of FC1 is *combined*
  together with the gradient of the routing probabilities.

Counterpart of the reference's MegaMoE / DeepEP path (``use_turbo_mega_moe``, ``use_turbo_deepep``:
primus/backends/megatron/core/extensions/primus_turbo.py:2331-2343, sync-free stages
primus/backends/megatron/patches/args/rocm_arg_validation.py:44-73).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import moe as moe_ops
from .symm_mem import SymmetricBuffer

COMM_CTAS = 20
BLOCK = 128


def _align(n: int, a: int = 4096) -> int:
    return -(-n // a) * a


@dataclass
class EPPlan:
    T: int
    k: int
    sched: moe_ops.Schedule          # padded layout of this rank's experts
    src_map: torch.Tensor            # [rows_cap] int32  (peer << 24 | token), -1 padding
    probs_perm: torch.Tensor         # [rows_cap] fp32 routing probability of every local row (0 for padding)
    pull_src: torch.Tensor           # [T*k] int32 (peer << 24 | row) in expert-sorted order of this rank's copies
    inv_order: torch.Tensor          # [T, k] int32 sorted position of copy (t, j)
    tok_sorted: torch.Tensor         # [T*k] int32 token of every sorted position


class FusedEP:
    """Symmetric workspace + launchers for one expert-parallel group and one problem shape."""

    def __init__(self, group, T: int, k: int, num_experts: int, hidden: int, capacity_factor: Optional[float] = None,
                 device: Optional[torch.device] = None):
        self.group = group
        self.ep = dist.get_world_size(group) if (dist.is_initialized() and group is not None) else 1
        self.rank = dist.get_rank(group) if (dist.is_initialized() and group is not None) else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.T, self.k, self.E, self.H = T, k, num_experts, hidden
        assert num_experts % self.ep == 0 and hidden % 8 == 0 and hidden * 2 <= 16384
        self.e_local = num_experts // self.ep
        factor = float(self.ep) if capacity_factor is None else min(float(capacity_factor), float(self.ep))
        self.rows_cap = moe_ops.rows_capacity(int(T * k * factor), self.e_local)
        self.num_mb = self.rows_cap // BLOCK
        ep, E, R = self.ep, self.E, self.rows_cap
        off = 0
        self.off = {}
        for name, nbytes in (("counts", ep * E * 4), ("src_map", R * 4), ("prob", R * 4), ("aux", R * 4),
                             ("ready", ep * self.num_mb * 4), ("x", T * hidden * 2), ("o", R * hidden * 2)):
            self.off[name] = off
            off += _align(nbytes)
        self.sym = SymmetricBuffer(off, group if self.ep > 1 else None, self.device)
        s = self.sym
        self.counts_all = s.local(torch.int32, ep * E, self.off["counts"])
        self.src_map_sym = s.local(torch.int32, R, self.off["src_map"])
        self.prob_sym = s.local(torch.float32, R, self.off["prob"])
        self.aux_sym = s.local(torch.float32, R, self.off["aux"])
        self.ready = s.local(torch.int32, ep * self.num_mb, self.off["ready"])
        self.x_sym = s.local(torch.bfloat16, T * hidden, self.off["x"]).view(T, hidden)
        self.o_sym = s.local(torch.bfloat16, R * hidden, self.off["o"]).view(R, hidden)

        def dev_table(name):
            return torch.tensor([s.peer_ptr(r, self.off[name]) for r in range(ep)], dtype=torch.int64, device=self.device)

        def host_table(name):
            return (ctypes.c_long * 8)(*[s.peer_ptr(r, self.off[name]) for r in range(ep)], *([0] * (8 - ep)))

        self.peer_counts_dev = dev_table("counts")
        self.peer_src_map_dev = dev_table("src_map")
        self.peer_prob_dev = dev_table("prob")
        self.peer_x = host_table("x")
        self.peer_o = host_table("o")
        self.peer_aux = host_table("aux")
        self.peer_ready = host_table("ready")
        self.gather_words = torch.zeros(self.num_mb, dtype=torch.int32, device=self.device)
        self.tile_words = torch.zeros(self.num_mb, dtype=torch.int32, device=self.device)
        self.n_seg = int(_lib.require().pb_moe_plan_num_segments(ctypes.c_int(T * k)))
        self.seg_counts = torch.zeros(self.n_seg * E, dtype=torch.int32, device=self.device)
        self.plan_scratch = torch.zeros(E + 1, dtype=torch.int32, device=self.device)
        self.gather_epoch = 0
        self.combine_epoch = 0
        self._published = False   # tokens of the current dispatch already ordered by the plan's barrier

    # ------------------------------------------------------------------ routing plan
    def plan(self, idx: torch.Tensor, probs: torch.Tensor) -> EPPlan:
        """idx [T, k] (any integer dtype), probs [T, k]; collective over the group, no host sync."""
        T, k = idx.shape
        assert T == self.T and k == self.k
        dev = self.device
        idx32 = idx.to(torch.int32).contiguous()
        p32 = probs.detach().float().contiguous()
        st = _lib.status_word(dev)
        _lib.call("moe_plan_count", idx32, T * k, self.E, self.ep, self.rank, self.seg_counts, self.plan_scratch,
                  self.peer_counts_dev, self.src_map_sym, self.rows_cap)
        self.sym.barrier()
        pull_src = torch.empty(T * k, dtype=torch.int32, device=dev)
        inv_order = torch.empty(T, k, dtype=torch.int32, device=dev)
        tok_sorted = torch.empty(T * k, dtype=torch.int32, device=dev)
        counts_local = torch.empty(self.e_local, dtype=torch.int32, device=dev)
        _lib.call("moe_plan_assign", idx32, p32, T * k, k, self.E, self.ep, self.rank, self.counts_all,
                  self.seg_counts, self.peer_src_map_dev, self.peer_prob_dev, self.rows_cap, pull_src, inv_order, tok_sorted,
                  counts_local, st)
        self._published = True   # the barrier above also separates the previous readers of x_sym from the next copy
        return _PendingPlan(self, T, k, counts_local, pull_src, inv_order, tok_sorted)

    # ------------------------------------------------------------------ kernels
    def _launch(self, gather: int, b_mn: int, A, B, D, N: int, K: int, sched, list_len: int, list_src, peer_src, dst,
                aux_dst=None):
        lib = _lib.require()
        fn = lib.pb_moe_fused
        fn.restype = ctypes.c_int
        vp, ci = ctypes.c_void_p, ctypes.c_int
        null = vp(0)
        if gather:
            self.gather_epoch += 1
            epoch, words = self.gather_epoch, self.gather_words
        else:
            self.combine_epoch += 1
            epoch, words = self.combine_epoch, self.tile_words
        _lib.LAUNCH_COUNT += 1
        rc = fn(ci(gather), ci(b_mn), ci(self.ep), ci(self.rank), ci(epoch), ci(COMM_CTAS), vp(A.data_ptr()),
                vp(B.data_ptr()), vp(D.data_ptr()), ci(self.rows_cap), ci(N), ci(K), ci(self.e_local),
                vp(sched.mblock_expert.data_ptr()), ci(list_len), vp(list_src.data_ptr()), peer_src, vp(dst.data_ptr()),
                self.peer_aux if aux_dst is not None else null,
                vp(aux_dst.data_ptr()) if aux_dst is not None else null, vp(words.data_ptr()),
                self.peer_ready if not gather else null, vp(self.ready.data_ptr()), ci(self.num_mb),
                vp(_lib.status_word(self.device).data_ptr()), _lib.stream_ptr())
        if rc != 0:
            raise _lib.NativeLibraryError(f"pb_moe_fused failed with code {rc}")

    def dispatch_gemm(self, x: torch.Tensor, w: torch.Tensor, plan: EPPlan, b_mn: bool):
        """Gathers this rank's expert rows from the owners' ``x`` [T, H] and multiplies them with the local
        expert weights.  Returns (gathered rows [rows_cap, H], product [rows_cap, N])."""
        assert x.shape == (self.T, self.H)
        if not self._published:
            self.sym.barrier()          # every peer has finished reading the previous contents of x_sym
        self._published = False
        self.x_sym.copy_(x)
        self.sym.barrier()              # tokens (and, after a plan, the source maps) are visible everywhere
        plan = plan.finalize() if isinstance(plan, _PendingPlan) else plan
        N = w.shape[2] if b_mn else w.shape[1]
        a_local = torch.empty(self.rows_cap, self.H, dtype=torch.bfloat16, device=self.device)
        out = torch.empty(self.rows_cap, N, dtype=torch.bfloat16, device=self.device)
        self._launch(1, int(b_mn), a_local, w, out, N, self.H, plan.sched, self.rows_cap, plan.src_map, self.peer_x,
                     a_local)
        return a_local, out

    def gemm_combine(self, a: torch.Tensor, w: torch.Tensor, plan: EPPlan, b_mn: bool, aux: Optional[torch.Tensor] = None):
        """Multiplies the local expert rows ``a`` [rows_cap, K] with the expert weights (output width H), lets
        every token owner pull its rows and sums the top-k copies.  Returns out [T, H] (and the gathered
        per-copy float [T, k] when ``aux`` [rows_cap] is given)."""
        plan = plan.finalize() if isinstance(plan, _PendingPlan) else plan
        K = a.shape[1]
        recv = torch.empty(self.T * self.k, self.H, dtype=torch.bfloat16, device=self.device)
        aux_out = None
        if aux is not None:
            self.aux_sym.copy_(aux)
            aux_out = torch.empty(self.T * self.k, dtype=torch.float32, device=self.device)
        self._launch(0, int(b_mn), a, w, self.o_sym, self.H, K, plan.sched, self.T * self.k, plan.pull_src, self.peer_o,
                     recv, aux_out)
        out = torch.empty(self.T, self.H, dtype=torch.bfloat16, device=self.device)
        _lib.call("moe_combine_rows", recv, plan.inv_order, out, self.T, self.k, self.H)
        if aux is not None:
            return out, aux_out[plan.inv_order.long().reshape(-1)].view(self.T, self.k)
        return out


class _PendingPlan:
    """A plan whose destination-side tables (source map, probabilities) become valid after the barrier that
    :meth:`FusedEP.dispatch_gemm` issues; ``finalize`` snapshots them once."""

    def __init__(self, ws: FusedEP, T, k, counts_local, pull_src, inv_order, tok_sorted):
        self.ws, self.T, self.k = ws, T, k
        self.counts_local, self.pull_src, self.inv_order, self.tok_sorted = counts_local, pull_src, inv_order, tok_sorted
        self._final: Optional[EPPlan] = None

    def finalize(self) -> EPPlan:
        if self._final is None:
            ws = self.ws
            sched = moe_ops.build_schedule(self.counts_local, ws.rows_cap)
            src_map = ws.src_map_sym.clone()
            probs_perm = torch.where(src_map >= 0, ws.prob_sym, torch.zeros_like(ws.prob_sym))
            self._final = EPPlan(self.T, self.k, sched, src_map, probs_perm, self.pull_src, self.inv_order,
                                 self.tok_sorted)
        return self._final


class _DispatchGemm1(torch.autograd.Function):
    """(x [T, H], probs [T, k], w1 [E_local, N, H]) -> (h1 [rows_cap, N], probs_perm [rows_cap])."""

    @staticmethod
    def forward(ctx, x, probs, w1, ws: FusedEP, plan):
        x_perm, h1 = ws.dispatch_gemm(x.contiguous(), w1, plan, False)
        fp = plan.finalize()
        ctx.save_for_backward(x_perm, w1)
        ctx.ws, ctx.plan, ctx.w_ref, ctx.probs_dtype = ws, fp, w1, probs.dtype
        return h1, fp.probs_perm.clone()

    @staticmethod
    def backward(ctx, dh1, dprobs_perm):
        x_perm, w1 = ctx.saved_tensors
        ws, plan = ctx.ws, ctx.plan
        dh1 = dh1.contiguous()
        dw = moe_ops.grouped_wgrad(dh1, x_perm, ctx.w_ref, plan.sched) if ctx.needs_input_grad[2] else None
        if dprobs_perm is None:
            dprobs_perm = torch.zeros(ws.rows_cap, dtype=torch.float32, device=dh1.device)
        dx, dprobs = ws.gemm_combine(dh1, w1, plan, True, aux=dprobs_perm.float().contiguous())
        return dx, dprobs.to(ctx.probs_dtype), dw, None, None


class _Gemm2Combine(torch.autograd.Function):
    """(act [rows_cap, I], w2 [E_local, H, I]) -> out [T, H] (sum over the top-k copies of every token)."""

    @staticmethod
    def forward(ctx, act, w2, ws: FusedEP, plan):
        out = ws.gemm_combine(act.contiguous(), w2, plan, False)
        ctx.save_for_backward(act, w2)
        ctx.ws, ctx.plan, ctx.w_ref = ws, plan.finalize(), w2
        return out

    @staticmethod
    def backward(ctx, dout):
        act, w2 = ctx.saved_tensors
        ws, plan = ctx.ws, ctx.plan
        dout_perm, dact = ws.dispatch_gemm(dout.contiguous(), w2, plan, True)
        dw = moe_ops.grouped_wgrad(dout_perm, act, ctx.w_ref, plan.sched) if ctx.needs_input_grad[1] else None
        return dact, dw, None, None


def dispatch_gemm1(x, probs, w1, ws, plan):
    return _DispatchGemm1.apply(x, probs, w1, ws, plan)


def gemm2_combine(act, w2, ws, plan):
    return _Gemm2Combine.apply(act, w2, ws, plan)


_WS: dict = {}


def get_workspace(group, T: int, k: int, num_experts: int, hidden: int, capacity_factor=None) -> FusedEP:
    key = (id(group), T, k, num_experts, hidden, capacity_factor)
    ws = _WS.get(key)
    if ws is None:
        ws = FusedEP(group, T, k, num_experts, hidden, capacity_factor)
        _WS[key] = ws
    return ws
