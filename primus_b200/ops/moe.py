"""MoE building blocks: router (score function, top-k, group-limited routing, expert bias, aux losses),
token permutation into the padded expert-major layout, grouped GEMMs, and the un-weighted top-k combine.

Semantics follow the reference's router and grouped MLP:
* router (primus/backends/megatron/core/transformer/moe/router.py:24-134): softmax before or after top-k,
  sigmoid scores with expert bias used for selection only, group-limited top-k, scaling factor, aux /
  sequence-aux load-balancing losses;
* expert MLP (primus/backends/megatron/core/transformer/experts.py:24-268): ``fc1 -> swiglu * routing
  prob -> fc2``; the probability multiplies the intermediate activation, so the combine after the
  expert computation is an un-weighted sum over the top-k copies.

Device-side scheduling: per-expert token counts never travel to the host in the single-rank path — the
padded row offsets and the row-block -> expert table are built by a kernel (``pb_moe_build_schedule``)
and consumed by the grouped GEMM (``csrc/grouped_gemm.cu``); buffers are sized for the worst case.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib

BLOCK_ROWS = 128


# ----------------------------------------------------------------------------------------------
# Router
class RouterFn(torch.autograd.Function):
    """Fused router (``csrc/router.cu``): logits [T, E] -> (probs [T, k] fp32, idx [T, k] int64, full [T, E] fp32,
    counts [E] int32)."""

    @staticmethod
    def forward(ctx, logits, bias, topk, sigmoid, pre_softmax, num_groups, group_topk, scale):
        T, E = logits.shape
        dev = logits.device
        lg = logits.contiguous()
        if lg.dtype not in (torch.bfloat16, torch.float32):
            lg = lg.float()
        probs = torch.empty(T, topk, dtype=torch.float32, device=dev)
        idx = torch.empty(T, topk, dtype=torch.int32, device=dev)
        full = torch.empty(T, E, dtype=torch.float32, device=dev)
        counts = torch.zeros(E, dtype=torch.int32, device=dev)
        b = bias.float().contiguous() if bias is not None else None
        _lib.call("router_fwd", lg, int(lg.dtype == torch.bfloat16), b, T, E, topk, int(sigmoid), int(pre_softmax),
                  int(num_groups or 0), int(group_topk or 0), float(scale), probs, idx, full, counts)
        ctx.save_for_backward(full, idx, probs)
        ctx.cfg = (topk, int(sigmoid), int(pre_softmax), float(scale), logits.dtype)
        idx64 = idx.long()
        ctx.mark_non_differentiable(idx64, counts)
        return probs, idx64, full, counts

    @staticmethod
    def backward(ctx, dprobs, _didx, dfull, _dcounts):
        full, idx, probs = ctx.saved_tensors
        topk, sigmoid, pre_softmax, scale, dt = ctx.cfg
        T, E = full.shape
        dlogits = torch.empty(T, E, dtype=torch.float32, device=full.device)
        dp = dprobs.float().contiguous() if dprobs is not None else torch.zeros_like(probs)
        df = dfull.float().contiguous() if dfull is not None else None
        _lib.call("router_bwd", dp, df, full, idx, probs, T, E, topk, sigmoid, pre_softmax, scale, dlogits)
        return dlogits.to(dt), None, None, None, None, None, None, None


def router_scores(logits: torch.Tensor, topk: int, score_function: str = "softmax", pre_softmax: bool = False,
                  expert_bias: Optional[torch.Tensor] = None, scaling_factor: Optional[float] = None,
                  num_groups: Optional[int] = None, group_topk: Optional[int] = None, return_counts: bool = False,
                  fixed_idx: Optional[torch.Tensor] = None):
    """Returns (probs [T, k] fp32, idx [T, k] int64, full scores [T, E] fp32 used by the aux losses) and, with
    ``return_counts``, the per-expert token counts (int32 [E]).  ``score_function`` "sqrtsoftplus" (DeepSeek-V4:
    ``sqrt(softplus(logit))``, handled like sigmoid scores) and ``fixed_idx`` (hash routing: the experts are given, only
    the weights come from the scores) run as composed PyTorch operations on every device."""
    if score_function not in ("softmax", "sigmoid", "sqrtsoftplus"):
        raise ValueError(f"unknown moe_router_score_function {score_function!r}")
    if logits.is_cuda and logits.shape[1] <= 1024 and topk <= 32 and fixed_idx is None and score_function != "sqrtsoftplus":
        probs, idx, full, counts = RouterFn.apply(logits, expert_bias, topk, score_function == "sigmoid", pre_softmax,
                                                  num_groups, group_topk, scaling_factor or 1.0)
        return (probs, idx, full, counts) if return_counts else (probs, idx, full)
    out = router_scores_ref(logits, topk, score_function, pre_softmax, expert_bias, scaling_factor, num_groups,
                            group_topk, fixed_idx)
    if return_counts:
        return (*out, torch.bincount(out[1].reshape(-1), minlength=logits.shape[1]).to(torch.int32))
    return out


def router_scores_ref(logits: torch.Tensor, topk: int, score_function: str = "softmax", pre_softmax: bool = False,
                      expert_bias: Optional[torch.Tensor] = None, scaling_factor: Optional[float] = None,
                      num_groups: Optional[int] = None, group_topk: Optional[int] = None,
                      fixed_idx: Optional[torch.Tensor] = None):
    """Plain PyTorch router (CPU path and numerics oracle of the fused kernel)."""
    lf = logits.float()
    T, E = lf.shape

    def select(scores_for_choice):
        if fixed_idx is not None:
            return fixed_idx.long()
        if num_groups and group_topk and num_groups > 1:
            g = scores_for_choice.view(T, num_groups, E // num_groups)
            gscore = g.topk(min(2, E // num_groups), dim=-1).values.sum(-1) if expert_bias is not None \
                else g.max(-1).values
            gidx = gscore.topk(group_topk, dim=-1).indices
            gmask = torch.zeros(T, num_groups, dtype=torch.bool, device=lf.device).scatter_(1, gidx, True)
            mask = gmask[:, :, None].expand(T, num_groups, E // num_groups).reshape(T, E)
            scores_for_choice = scores_for_choice.masked_fill(~mask, float("-inf"))
        return scores_for_choice.topk(topk, dim=-1).indices

    if score_function == "softmax":
        if pre_softmax:
            full = torch.softmax(lf, dim=-1)
            idx = select(full)
            probs = full.gather(1, idx)
        else:
            full = torch.softmax(lf, dim=-1)
            idx = select(lf)
            probs = torch.softmax(lf.gather(1, idx), dim=-1)
    elif score_function in ("sigmoid", "sqrtsoftplus"):
        full = torch.sigmoid(lf) if score_function == "sigmoid" else torch.sqrt(torch.nn.functional.softplus(lf))
        choice = full + expert_bias.float()[None, :] if expert_bias is not None else full
        idx = select(choice)
        probs = full.gather(1, idx)
        if topk > 1:
            probs = probs / (probs.sum(-1, keepdim=True) + 1e-20)
    else:
        raise ValueError(f"unknown moe_router_score_function {score_function!r}")
    if scaling_factor:
        probs = probs * scaling_factor
    return probs, idx, full


def load_balancing_loss(full_scores: torch.Tensor, idx: torch.Tensor, num_experts: int, topk: int, coeff: float,
                        seq_len: Optional[int] = None) -> torch.Tensor:
    """Switch-style aux loss ``coeff * E * sum_e f_e * P_e`` with ``f_e`` the fraction of routed tokens and
    ``P_e`` the mean score.  With ``seq_len`` the loss is computed per sequence and averaged
    (``seq_aux_loss``)."""
    T, E = full_scores.shape
    if seq_len:
        B = T // seq_len
        scores = full_scores.view(B, seq_len, E)
        onehot = torch.zeros(B, seq_len, E, device=idx.device, dtype=torch.float32)
        onehot.scatter_(2, idx.view(B, seq_len, topk), 1.0)
        f = onehot.sum(1) / (seq_len * topk)
        P = scores.mean(1)
        return coeff * E * (f * P).sum(-1).mean()
    counts = torch.bincount(idx.reshape(-1), minlength=E).float()
    f = counts / (T * topk)
    P = full_scores.mean(0)
    return coeff * E * (f * P).sum()


# ----------------------------------------------------------------------------------------------
# Schedule + permutation
class Schedule:
    """Padded expert-major layout of the routed token copies of one rank."""

    def __init__(self, counts, padded, row_start, mblock_expert, total_rows, rows_cap):
        self.counts, self.padded, self.row_start = counts, padded, row_start
        self.mblock_expert, self.total_rows, self.rows_cap = mblock_expert, total_rows, rows_cap


def rows_capacity(num_copies: int, num_experts: int) -> int:
    """Worst-case padded row count for ``num_copies`` routed rows over ``num_experts`` experts."""
    cap = num_copies + num_experts * (BLOCK_ROWS - 1)
    return -(-cap // BLOCK_ROWS) * BLOCK_ROWS


def build_schedule(counts: torch.Tensor, rows_cap: int) -> Schedule:
    """counts: int32 [E] tokens per (local) expert."""
    E = counts.numel()
    dev = counts.device
    max_mb = rows_cap // BLOCK_ROWS
    if counts.is_cuda:
        padded = torch.empty(E, dtype=torch.int32, device=dev)
        row_start = torch.empty(E, dtype=torch.int32, device=dev)
        mblock_expert = torch.empty(max_mb, dtype=torch.int32, device=dev)
        total = torch.empty(1, dtype=torch.int32, device=dev)
        _lib.call("moe_build_schedule", counts, E, max_mb, padded, row_start, mblock_expert, total)
    else:
        padded = ((counts + BLOCK_ROWS - 1) // BLOCK_ROWS * BLOCK_ROWS).to(torch.int32)
        row_start = (torch.cumsum(padded, 0) - padded).to(torch.int32)
        total = padded.sum().reshape(1).to(torch.int32)
        mb_start = torch.arange(max_mb, dtype=torch.int32) * BLOCK_ROWS
        ends = torch.cumsum(padded, 0)
        e = torch.searchsorted(ends, mb_start, right=True).to(torch.int32)
        mblock_expert = torch.where(mb_start < total, e, torch.full_like(e, -1))
    return Schedule(counts, padded, row_start, mblock_expert, total, rows_cap)


def permutation_maps(expert_of_copy: torch.Tensor, sched: Schedule):
    """expert_of_copy: int64 [R] local expert of every routed row (in arrival order).
    Returns (src [rows_cap] int32: arrival row feeding each padded row, -1 for padding;
             pos [R] int32: padded row of every arrival row)."""
    R = expert_of_copy.numel()
    dev = expert_of_copy.device
    order = torch.argsort(expert_of_copy, stable=True)
    sorted_e = expert_of_copy[order]
    cum = torch.cumsum(sched.counts.long(), 0) - sched.counts.long()
    rank_in_e = torch.arange(R, device=dev) - cum[sorted_e]
    dest = sched.row_start.long()[sorted_e] + rank_in_e
    src = torch.full((sched.rows_cap,), -1, dtype=torch.int32, device=dev)
    src[dest] = order.to(torch.int32)
    pos = torch.empty(R, dtype=torch.int32, device=dev)
    pos[order] = dest.to(torch.int32)
    return src, pos


class GatherRowsFn(torch.autograd.Function):
    """out[r] = x[src[r]] (zero rows where src < 0). Backward: dx[t] = sum over the rows fed by t."""

    @staticmethod
    def forward(ctx, x, src, inv_pos, total_rows):
        R = src.numel()
        H = x.shape[-1]
        out = torch.empty(R, H, dtype=x.dtype, device=x.device)
        _lib.call("moe_gather_rows", x, src, None, out, R, H, None)
        ctx.save_for_backward(inv_pos)
        ctx.T = x.shape[0]
        return out

    @staticmethod
    def backward(ctx, dout):
        (inv_pos,) = ctx.saved_tensors
        T = ctx.T
        k = inv_pos.numel() // T
        H = dout.shape[-1]
        dx = torch.empty(T, H, dtype=dout.dtype, device=dout.device)
        _lib.call("moe_combine_rows", dout.contiguous(), inv_pos, dx, T, k, H)
        return dx, None, None, None


class CombineRowsFn(torch.autograd.Function):
    """out[t] = sum_k y[pos[t, k]]. Backward: dy[r] = dout[token of r] (zero for padding rows)."""

    @staticmethod
    def forward(ctx, y, pos, src_token):
        T, k = pos.shape
        H = y.shape[-1]
        out = torch.empty(T, H, dtype=y.dtype, device=y.device)
        _lib.call("moe_combine_rows", y, pos.contiguous(), out, T, k, H)
        ctx.save_for_backward(src_token)
        ctx.R = y.shape[0]
        return out

    @staticmethod
    def backward(ctx, dout):
        (src_token,) = ctx.saved_tensors
        H = dout.shape[-1]
        dy = torch.empty(ctx.R, H, dtype=dout.dtype, device=dout.device)
        _lib.call("moe_gather_rows", dout.contiguous(), src_token, None, dy, ctx.R, H, None)
        return dy, None, None


def gather_rows(x, src, inv_pos):
    """x [T, H] -> [rows_cap, H]; ``inv_pos`` [T, k] are the padded rows fed by each token (for backward)."""
    if not x.is_cuda:
        out = x.new_zeros(src.numel(), x.shape[-1])
        m = src >= 0
        out[m] = x[src[m].long()]
        return out
    return GatherRowsFn.apply(x, src, inv_pos, None)


def combine_rows(y, pos, src_token):
    """y [rows_cap, H], pos [T, k] -> [T, H] un-weighted sum; ``src_token`` [rows_cap] token of each row."""
    if not y.is_cuda:
        T, k = pos.shape
        g = y[pos.clamp_min(0).long().reshape(-1)].view(T, k, -1)
        g = g * (pos >= 0).unsqueeze(-1).to(g.dtype)
        return g.sum(1)
    return CombineRowsFn.apply(y, pos, src_token)


# ----------------------------------------------------------------------------------------------
# Grouped GEMM
def _grouped_ref(x, w, sched: Schedule, trans_w: bool):
    out = x.new_zeros(x.shape[0], w.shape[2] if trans_w else w.shape[1])
    rs, pd = sched.row_start.tolist(), sched.padded.tolist()
    for e in range(w.shape[0]):
        if pd[e]:
            xe = x[rs[e]:rs[e] + pd[e]].float()
            we = w[e].float()
            out[rs[e]:rs[e] + pd[e]] = (xe @ (we if trans_w else we.t())).to(x.dtype)
    return out


_EXPERT_W_CACHE: dict = {}


def _grouped_fp8_eligible(x, w) -> bool:
    """MXFP8 grouped GEMMs need the recipe switched on and every dimension a multiple of 128."""
    from . import gemm

    if not x.is_cuda or gemm.fp8_recipe() is None or getattr(w, "_fp8_exempt", False):
        return False
    E, N, K = w.shape
    return x.shape[0] % 128 == 0 and N % 128 == 0 and K % 128 == 0 and x.dtype == torch.bfloat16


def _quantized_expert_weight(w):
    """Both MXFP8 directions of an expert weight [E, N, K] (quantised as the [E*N, K] matrix: blocks never straddle
    experts because N is a multiple of 128), cached until the optimizer next changes the parameters."""
    from . import fp8, gemm

    gen = gemm.weight_generation()
    hit = _EXPERT_W_CACHE.get(id(w))
    if hit is None or hit[0] != gen or hit[1] != w.data_ptr():
        E, N, K = w.shape
        hit = (gen, w.data_ptr(), fp8.quantize_mxfp8(w.detach().view(E * N, K), True, True, is_weight=True,
                                                         slot_key=(id(w), "w")))
        _EXPERT_W_CACHE[id(w)] = hit
    return hit[2]


def grouped_wgrad(dy, x, w, sched: Schedule, dyq=None):
    """dW[e] = dy_e^T x_e over the rows of expert e.  Accumulates into ``w.main_grad`` (fp32) when the parameter
    has one (returns None and fires the bucket callback), else returns the gradient in ``w.dtype``.
    ``dyq``: the MXFP8 copy of ``dy`` (column direction) when the caller already has one; the MXFP8 path is taken when
    the recipe is on and the shapes allow it."""
    E, N, K = w.shape
    mg = getattr(w, "main_grad", None)
    tgt = mg if mg is not None else torch.empty(E, N, K, dtype=torch.float32, device=x.device)
    if _grouped_fp8_eligible(x, w) and dy.shape[0] % 128 == 0:
        from . import fp8

        if dyq is None or dyq.q_col is None:
            dyq = fp8.quantize_mxfp8(dy.contiguous(), False, True, slot_key=(id(w), "dy"))
        xq = fp8.quantize_mxfp8(x, False, True, slot_key=(id(w), "x"))
        _lib.call("grouped_gemm_mxfp8", 2, dyq.q_col, dyq.sf_col, xq.q_col, xq.sf_col, tgt, x.shape[0], N, K, E,
                  sched.mblock_expert, sched.row_start, sched.padded, int(mg is not None), _lib.status_word(x.device))
    else:
        _lib.call("grouped_gemm", 2, dy, x, tgt, x.shape[0], N, K, E, sched.mblock_expert, sched.row_start,
                  sched.padded, int(mg is not None), _lib.status_word(x.device))
    if mg is None:
        return tgt.to(w.dtype)
    cb = getattr(w, "_grad_ready_cb", None)
    if cb is not None:
        cb(w)
    return None


class GroupedLinearFn(torch.autograd.Function):
    """y[rows of e] = x[rows of e] @ w[e]^T with w [E, N, K]; dW accumulates into ``w.main_grad`` when present."""

    @staticmethod
    def forward(ctx, x, w, sched: Schedule):
        E, N, K = w.shape
        out = torch.empty(x.shape[0], N, dtype=x.dtype, device=x.device)
        ctx.fp8 = _grouped_fp8_eligible(x, w)
        if ctx.fp8:
            from . import fp8

            xq = fp8.quantize_mxfp8(x, True, False, slot_key=(id(w), "x"))
            wq = _quantized_expert_weight(w)
            _lib.call("grouped_gemm_mxfp8", 0, xq.q_row, xq.sf_row, wq.q_row, wq.sf_row, out, x.shape[0], N, K, E,
                      sched.mblock_expert, sched.row_start, sched.padded, 0, _lib.status_word(x.device))
        else:
            _lib.call("grouped_gemm", 0, x, w, out, x.shape[0], N, K, E, sched.mblock_expert, sched.row_start,
                      sched.padded, 0, _lib.status_word(x.device))
        ctx.save_for_backward(x, w)
        ctx.sched = sched
        ctx.w_ref = w
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        sched = ctx.sched
        E, N, K = w.shape
        dy = dy.contiguous()
        dx = None
        if ctx.fp8:
            from . import fp8

            dyq = fp8.quantize_mxfp8(dy, ctx.needs_input_grad[0], ctx.needs_input_grad[1], slot_key=(id(w), "dy"))
            if ctx.needs_input_grad[0]:
                wq = _quantized_expert_weight(w)
                dx = torch.empty_like(x)
                _lib.call("grouped_gemm_mxfp8", 1, dyq.q_row, dyq.sf_row, wq.q_col, wq.sf_col, dx, x.shape[0], K, N, E,
                          sched.mblock_expert, sched.row_start, sched.padded, 0, _lib.status_word(x.device))
            dw = grouped_wgrad(dy, x, ctx.w_ref, sched, dyq=dyq) if ctx.needs_input_grad[1] else None
            return dx, dw, None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            _lib.call("grouped_gemm", 1, dy, w, dx, x.shape[0], K, N, E, sched.mblock_expert, sched.row_start,
                      sched.padded, 0, _lib.status_word(x.device))
        dw = grouped_wgrad(dy, x, ctx.w_ref, sched) if ctx.needs_input_grad[1] else None
        return dx, dw, None


def grouped_linear(x, w, sched: Schedule):
    if not x.is_cuda:
        return _GroupedRefFn.apply(x, w, sched)
    return GroupedLinearFn.apply(x, w, sched)


class _GroupedRefFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, sched):
        ctx.save_for_backward(x, w)
        ctx.sched = sched
        return _grouped_ref(x, w, sched, False)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        s = ctx.sched
        dx = _grouped_ref(dy, w, s, True)
        dw = torch.zeros_like(w, dtype=torch.float32)
        rs, pd = s.row_start.tolist(), s.padded.tolist()
        for e in range(w.shape[0]):
            if pd[e]:
                dw[e] = dy[rs[e]:rs[e] + pd[e]].float().t() @ x[rs[e]:rs[e] + pd[e]].float()
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            mg.add_(dw)
            return dx, None, None
        return dx, dw.to(w.dtype), None
